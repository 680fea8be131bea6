#!/usr/bin/env python
"""Benchmark of the Qwen3 training hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is a full training step (forward, backward, AdamW step) of a random-init
Qwen3-8B-shaped model (36 layers, hidden 4096, 32/8 heads, head_dim 128,
intermediate 12288, vocab 151936, bf16) on one sequence of 8192 synthetic tokens,
with RMSNorm, RoPE, the SwiGLU MLP and the fused lm_head + cross-entropy running on
the bastile_b200 kernels and the optimizer step on bastile_b200.optim (--optimizer torch
selects torch.optim.AdamW as in the reference's own benchmark,
tests/benchmarks/e2e/qwen_8b_seqlen.py:80-203); attention and the products of the q/k/v/o
projections are stock PyTorch (cuDNN, cuBLAS).  By default the patch set is
`apply(fused_layers=True)` (residual adds folded into the norm / down-projection kernels,
q/k-norm + RoPE as one kernel, the q/k/v input gradient accumulated by the projection GEMMs;
--no-fused-layers for exactly the reference's four patches) and, on one GPU, the optimizer updates each large parameter
underneath the backward pass as soon as its gradient is complete (--no-overlap-optimizer).

With N > 1 (launched by torchrun, one rank per GPU) every rank steps its own sequence: weak
scaling by tokens.  --parallel selects how the ranks cooperate:
  sharded  (default) bastile_b200.optim.ShardedAdamW: gradients reduce-scattered per bucket over
           NCCL while the backward pass still runs, AdamW on this rank's 1/N of every bucket,
           parameters all-gathered in place;
  ddp      DistributedDataParallel + the AdamW step after the backward pass;
  fsdp, fsdp-vp  FullyShardedDataParallel FULL_SHARD per decoder layer (the reference's
           tests/benchmarks/e2e/qwen_8b_fsdp.py:161-168), with -vp the lm_head rows sharded over
           the ranks and the fused loss run vocabulary-parallel.

Rank 0 prints ONE JSON line.  `value` is tokens/s with the step's inputs already on
the device; `e2e` is the same loop fed from pinned host buffers with the loss read
back every step.  `roofline` describes the dominant kernel (the tcgen05 GEMM that
runs the MLP block) from CUDA events recorded around its launches inside the timed
steps.  At N = 1 the line also carries `per_op` (forward+backward micro-benchmarks of the ops at
the per-op benchmark shapes), `seq_sweep`, `comparators` (HF eager and Liger on the same GPU, as
in the reference's own benchmark) and `cpu_baseline` (HF eager on the host cores, bounded sample).
At N > 1 it carries `per_op` for the vocabulary-parallel fused loss with `vp_parity` (a self-check
against the unsharded op on the same inputs; a mismatch makes the run exit non-zero), `ddp` (the
same step under DistributedDataParallel, with the losses of both compared) and `sharded` (FSDP +
vocabulary-parallel loss at 8192 and 32768 tokens per rank).  `--impl reference` prints the CPU
measurement as its own line.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SEQ_LEN = 8192
QWEN3_8B = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6,
                rope_theta=1e6, tie_word_embeddings=False, max_position_embeddings=40960,
                attention_dropout=0.0, use_cache=False)
METRIC = "Qwen3-8B train tokens/s/B200"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# reference README bar chart (other GPU software stack, intermediate 14336): context only
REFERENCE_CHART = {"bastile_tokens_per_s_seq8192": 12.0e3, "bastile_over_pytorch": 1.24, "bastile_over_liger": 1.165}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """nvidia-smi samples of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()
        return False

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm),
                "sm_mhz_highest_seen": sm[-1]}


# ------------------------------------------------------------------- CPU baseline
def cpu_reference_sample(seq: int = 256, threads: int | None = None):
    """HF eager (unpatched) Qwen3 on the host cores, fp32, assembled from three timed pieces with
    Qwen3-8B shapes at `seq` tokens, each run once untimed first so that page faults of fresh
    allocations are not billed:
      A  one Qwen3DecoderLayer forward+backward (RMSNorm x4, RoPE, attention, SwiGLU MLP),
      B  final RMSNorm + lm_head + shifted cross-entropy forward+backward,
      C  torch.optim.AdamW step over the layer's parameters, scaled to the full parameter count.
    A 36-layer training step is 36*A + B + C*(P_model/P_layer).  Returns tokens/s."""
    import torch
    import torch.nn.functional as F
    import transformers.models.qwen3.modeling_qwen3 as q3
    from transformers import Qwen3Config

    import bastile_b200

    bastile_b200.reset()  # the path the patches replace: HF eager
    if threads is None:
        # torchrun exports OMP_NUM_THREADS=1; the CPU arm should use every core it may run on
        try:
            threads = len(os.sched_getaffinity(0))
        except AttributeError:
            threads = os.cpu_count() or 1
    if threads and threads != torch.get_num_threads():
        torch.set_num_threads(threads)
    cfg = Qwen3Config(**QWEN3_8B)
    cfg._attn_implementation = "sdpa"
    torch.manual_seed(0)
    hdim, vocab, layers = cfg.hidden_size, cfg.vocab_size, cfg.num_hidden_layers

    def timed_second(fn):
        fn()
        t0 = time.perf_counter()
        fn()
        return time.perf_counter() - t0

    layer = q3.Qwen3DecoderLayer(cfg, 0).float().train()
    rotary = q3.Qwen3RotaryEmbedding(cfg)
    x = torch.randn(1, seq, hdim, requires_grad=True)
    pos = torch.arange(seq)[None]
    dy = torch.randn(1, seq, hdim)

    def piece_a():
        for p in layer.parameters():
            p.grad = None
        x.grad = None
        out = layer(x, attention_mask=None, position_ids=pos, position_embeddings=rotary(x, pos))
        out = out[0] if isinstance(out, tuple) else out
        out.backward(dy)

    t_a = timed_second(piece_a)
    opt = torch.optim.AdamW(layer.parameters(), lr=1e-4)
    t_c = timed_second(opt.step)
    p_layer = sum(p.numel() for p in layer.parameters())
    del opt, layer

    norm = q3.Qwen3RMSNorm(hdim, eps=cfg.rms_norm_eps)
    head = torch.nn.Linear(hdim, vocab, bias=False)
    ids = torch.randint(0, vocab, (1, seq))

    def piece_b():
        head.weight.grad = norm.weight.grad = x.grad = None
        logits = head(norm(x)).float()
        loss = F.cross_entropy(logits[:, :-1].reshape(-1, vocab), ids[:, 1:].reshape(-1), ignore_index=-100)
        loss.backward()

    t_b = timed_second(piece_b)
    del head
    p_model = layers * p_layer + 2 * vocab * hdim + hdim
    t_step = layers * t_a + t_b + t_c * (p_model / p_layer)
    times = {"layer_fwd_bwd_s": t_a, "head_loss_fwd_bwd_s": t_b, "adamw_layer_s": t_c, "step36_s": t_step}
    return seq / t_step, times, torch.get_num_threads()


def run_reference_arm(args):
    """`--impl reference`: the path's CPU implementation (HF eager) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    seq = 256
    vals, walls = [], []
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_reference_sample(seq)
    t_begin = time.perf_counter()
    for _ in range(max(1, args.steps)):
        t0 = time.perf_counter()
        v, times, threads = cpu_reference_sample(seq)
        walls.append(time.perf_counter() - t0)
        vals.append(v)
        if time.perf_counter() - t_begin > 240:  # stay within a few minutes whatever K is
            break
    vals.sort()
    walls.sort()
    value = vals[len(vals) // 2]
    sample = (f"HF transformers eager Qwen3 (what bastile.reset() restores), fp32, Qwen3-8B shapes at {seq} tokens: "
              f"36 x (decoder layer fwd+bwd) + (final norm + lm_head + cross-entropy fwd+bwd) + AdamW scaled to 8.19 B "
              f"parameters; median of {len(vals)} samples; last: {json.dumps({k: round(v, 3) for k, v in times.items()})}")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": len(vals), "warmup": min(args.warmup, 1), "ms_per_step": SEQ_LEN / value * 1e3,
            "extrapolated": True,
            "ms_per_step_sample": walls[len(walls) // 2] * 1e3,
            "extrapolation": "ms_per_step is the time a full 8192-token, 36-layer step would take at the sampled rate "
                             "(it is NOT run: hours on these cores); ms_per_step_sample is the wall time of one sample "
                             "as actually executed (one layer + head/loss + one layer's AdamW at 256 tokens, each run "
                             "twice, model construction included)",
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"qwen3-8b ({QWEN3_8B['num_hidden_layers']} layers, hidden 4096, intermediate "
                                   f"{QWEN3_8B['intermediate_size']}, vocab 151936) seq {SEQ_LEN} batch 1 fwd+bwd+AdamW, "
                                   "random init",
                       "sample": f"bounded CPU sample at {seq} tokens, composed to a 36-layer step (see cpu_baseline)",
                       "global_batch_tokens": SEQ_LEN, "seq_len": SEQ_LEN, "parallelism": "host CPU threads"},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "reference",
                             "sample": sample},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "host_cpus": os.cpu_count(), "torch_threads": torch.get_num_threads()}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ per-op microbench
def _kernel_ms(fn, flush, iters, warm):
    """Median over `iters` calls of the device time spent inside the library calls that `fn`
    makes (CUDA events recorded around each call on its stream), L2 flushed before every call.
    The flush READS a 256 MiB buffer: it evicts what the previous call left without filling the
    L2 with dirty lines, whose write-back (up to 126 MB, about 20 us) a write-flush would charge
    to the first timed kernel."""
    import torch

    from bastile_b200 import _lib

    for _ in range(warm):
        fn()
    per_iter = []
    for _ in range(iters):
        flush.sum()  # streams 256 MiB (> 126 MB L2) through the cache, leaving clean lines
        torch.cuda._sleep(600_000)  # keep the GPU busy while the host queues the op, so that the
        # events bracket kernels that are already waiting in the stream (no host gaps inside)
        _lib.instr.reset(enabled=True)
        fn()
        per_iter.append(sum(ms for _, ms in _lib.instr.elapsed_ms().values()))
    _lib.instr.reset(enabled=False)
    per_iter.sort()
    return per_iter[len(per_iter) // 2]


def _hbm(ms, byts, peaks):
    g = byts / ms / 1e6
    return {"ms": ms, "GBps": g, "frac_of_hbm_peak": g / peaks["hbm_gbs"], "algorithmic_MB": byts / 1e6}


def _tensor(ms, flops, peaks):
    t = flops / ms / 1e9
    return {"ms": ms, "TFLOPs": t, "frac_of_bf16_burst": t / peaks["bf16_tflops"],
            "frac_of_bf16_sustained": t / peaks["bf16_tflops_sustained"], "algorithmic_TFLOP": flops / 1e12}


def _lce_inputs(dev, rows=16384, hdim=4096, vocab=151936, full_weight=False, rank=0, world=1):
    """Config-3 inputs, identical on every rank: hidden ~ N(0,1), labels uniform with 5 % ignored,
    lm_head ~ N(0, 0.02) (the whole matrix, or this rank's rows of it)."""
    import torch

    bf = torch.bfloat16
    gen = torch.Generator(device=dev).manual_seed(1)
    hid = torch.randn(rows, hdim, device=dev, dtype=bf, generator=gen)
    lab = torch.randint(0, vocab, (rows,), device=dev, generator=gen)
    lab[torch.rand(rows, device=dev, generator=gen) < 0.05] = -100
    w = torch.randn(vocab, hdim, device=dev, dtype=bf, generator=gen) * 0.02
    if not full_weight:
        vloc = vocab // world
        w = w[rank * vloc:(rank + 1) * vloc].clone()
    return hid, lab, w


def per_op_bench(peaks, only=None, iters=None, rows=None, lce_chunk=None):
    """Forward+backward of each op at the per-op benchmark shapes (bf16, seed 1), called through
    the public ops; the time is that of the kernels (events around the library calls).  `rows`
    shrinks the token count of the MLP block / fused loss (small cases for profiler captures)."""
    import torch

    from bastile_b200.ops.fused_linear_cross_entropy import fused_linear_cross_entropy
    from bastile_b200.ops.rms_norm import rms_norm
    from bastile_b200.ops.rope import RoPEFunction
    from bastile_b200.ops.swiglu import SwiGLUMLPFunction, swiglu

    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(1)
    flush = torch.zeros(64 << 20, dtype=torch.int32, device=dev)  # 256 MiB
    out = {}
    bf = torch.bfloat16
    want = lambda name: only is None or only == name  # noqa: E731

    def hbm_entry(make, run, byts, n_iters):
        """Two timings of one forward+backward: per call (events around each library call, L2 flushed
        before, launch latency of two short kernels included) and back to back (six independent
        input sets, far more than L2 together, queued behind a sleep kernel so that the launches
        are already waiting: kernel time without the per-call latency)."""
        sets = [make() for _ in range(6)]
        entry = _hbm(_kernel_ms(lambda: run(sets[0]), flush, n_iters, 5), byts, peaks)
        for t in sets:
            run(t)
        per_set = []
        for _ in range(5):
            torch.cuda.synchronize()
            torch.cuda._sleep(6_000_000)  # ~3 ms: the host queues all twelve launches meanwhile
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for t in sets:
                run(t)
            e1.record()
            torch.cuda.synchronize()
            per_set.append(e0.elapsed_time(e1) / len(sets))
        per_set.sort()
        ms_b = per_set[len(per_set) // 2]
        entry.update(ms_back_to_back=ms_b, GBps_back_to_back=byts / ms_b / 1e6,
                     frac_of_hbm_peak_back_to_back=byts / ms_b / 1e6 / peaks["hbm_gbs"])
        return entry

    if want("rmsnorm"):
        for m, n in ((8192, 4096), (262144, 128)):
            def make(m=m, n=n):
                return (torch.randn(m, n, device=dev, dtype=bf).requires_grad_(True),
                        (1 + 0.02 * torch.randn(n, device=dev)).to(bf).requires_grad_(True),
                        torch.randn(m, n, device=dev, dtype=bf))

            def rms(t):
                x, w, dy = t
                x.grad = w.grad = None
                rms_norm(x, w, 1e-6).backward(dy)

            out[f"rmsnorm_{m}x{n}_fwd_bwd"] = hbm_entry(make, rms, 5 * m * n * 2 + 8 * m + 6 * n, iters or 20)

    if want("rmsnorm"):
        from bastile_b200.ops.fused_layers import add_rms_norm

        m, n = 8192, 4096

        def make_add():
            return (torch.randn(m, n, device=dev, dtype=bf).requires_grad_(True), torch.randn(m, n, device=dev, dtype=bf),
                    (1 + 0.02 * torch.randn(n, device=dev)).to(bf).requires_grad_(True),
                    torch.randn(m, n, device=dev, dtype=bf), torch.randn(m, n, device=dev, dtype=bf))

        def add_rms(t):
            x, r, w, dy, ds = t
            x.grad = w.grad = None
            y, stream = add_rms_norm(x, r, w, 1e-6)
            torch.autograd.backward([y, stream], [dy, ds])

        # fwd: x, residual in; sum, y out.  bwd: dy, sum, d(stream) in; dx out.
        out[f"add_rmsnorm_{m}x{n}_fwd_bwd"] = hbm_entry(make_add, add_rms, 8 * m * n * 2 + 8 * m + 6 * n, iters or 20)

    if want("rope"):
        from bastile_b200.ops.fused_layers import qk_norm_rope as fused_qk

        inv = 1.0 / (1e6 ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128))
        emb = torch.outer(torch.arange(8192, dtype=torch.float32), inv)
        emb = torch.cat((emb, emb), -1)
        cos, sin = emb.cos()[None].to(dev, bf), emb.sin()[None].to(dev, bf)

        def make_qk():
            xq = torch.randn(1, 8192, 32, 128, device=dev, dtype=bf).requires_grad_(True)
            xk = torch.randn(1, 8192, 8, 128, device=dev, dtype=bf).requires_grad_(True)
            return (xq, xk, torch.ones(128, device=dev, dtype=bf, requires_grad=True),
                    torch.ones(128, device=dev, dtype=bf, requires_grad=True), torch.randn_like(xq), torch.randn_like(xk))

        def qk_norm_rope(t):
            xq, xk, wq, wk, dq, dk = t
            xq.grad = xk.grad = wq.grad = wk.grad = None
            qo, ko = fused_qk(xq, xk, wq, wk, cos, sin)
            torch.autograd.backward([qo, ko], [dq, dk])

        # fwd: heads in, heads out; bwd: d(out), heads in, d(heads) out; plus the cos/sin half rows
        byts = 5 * (8192 * 40 * 128) * 2 + 2 * 2 * 8192 * 64 * 2
        out["qk_norm_rope_q32_k8_8192x128_fwd_bwd"] = hbm_entry(make_qk, qk_norm_rope, byts, iters or 20)

        def make_rope():
            q = torch.randn(1, 32, 8192, 128, device=dev, dtype=bf).requires_grad_(True)
            k = torch.randn(1, 8, 8192, 128, device=dev, dtype=bf).requires_grad_(True)
            return q, k, torch.randn_like(q), torch.randn_like(k)

        def rope(t):
            q, k, dq, dk = t
            q.grad = k.grad = None
            qo, ko = RoPEFunction.apply(q * 1, k * 1, cos, sin)  # `* 1`: the op rotates its input in place
            torch.autograd.backward([qo, ko], [dq, dk])

        out["rope_q32_k8_8192x128_fwd_bwd"] = hbm_entry(make_rope, rope, 339.74e6, iters or 20)
        out["rope_q32_k8_8192x128_fwd_bwd"]["back_to_back_note"] = (
            "the back-to-back figure of this entry also contains the two `* 1` copies that keep the in-place op "
            "from rotating its own input twice (torch kernels, 2 x 168 MB)")

    if want("swiglu"):
        m, n = 8192, 12288

        def make_swi():
            return (torch.randn(m, n, device=dev, dtype=bf).requires_grad_(True),
                    torch.randn(m, n, device=dev, dtype=bf).requires_grad_(True), torch.randn(m, n, device=dev, dtype=bf))

        def swi(t):
            g, u, dh = t
            g.grad = u.grad = None
            swiglu(g, u).backward(dh)

        # fwd: gate, up in, h out; bwd: dh, gate, up in, dgate, dup out
        out[f"swiglu_elementwise_{m}x{n}_fwd_bwd"] = hbm_entry(make_swi, swi, 8 * m * n * 2, iters or 20)

    if want("adamw"):
        from bastile_b200.optim import AdamW as OurAdamW

        m, n = 12288, 4096  # one gate / up projection weight

        def make_adam():
            w = torch.nn.Parameter((torch.randn(m, n, device=dev) * 0.02).to(bf))
            w.grad = (torch.randn(m, n, device=dev) * 1e-3).to(bf)
            opt_w = OurAdamW([w], lr=1e-4)
            opt_w.step()  # creates the moments
            return w, opt_w

        def adam(t):
            t[1].step()

        # parameter, both moments: read and written; gradient: read (bf16 everything)
        out[f"adamw_{m}x{n}_step"] = hbm_entry(make_adam, adam, 7 * m * n * 2, iters or 20)

    if want("mlp"):
        t_mlp = rows or 8192
        xm = torch.randn(t_mlp, 4096, device=dev, dtype=bf).requires_grad_(True)
        wg = (torch.randn(12288, 4096, device=dev) * 0.02).to(bf).requires_grad_(True)
        wu = (torch.randn(12288, 4096, device=dev) * 0.02).to(bf).requires_grad_(True)
        wd = (torch.randn(4096, 12288, device=dev) * 0.02).to(bf).requires_grad_(True)
        dym = torch.randn(t_mlp, 4096, device=dev, dtype=bf)

        def mlp():
            xm.grad = wg.grad = wu.grad = wd.grad = None
            SwiGLUMLPFunction.apply(xm, wg, wu, wd).backward(dym)

        out[f"swiglu_mlp_{t_mlp}x4096x12288_fwd_bwd"] = _tensor(_kernel_ms(mlp, flush, iters or 10, 3),
                                                                7.4217e12 * t_mlp / 8192, peaks)
        del xm, wg, wu, wd, dym

    if want("lce"):
        import torch.distributed as dist

        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        vloc = 151936 // world  # 75968 / 37984 / 18992 rows of lm_head per rank at 2 / 4 / 8 GPUs
        t_lce = rows or 16384
        hid, lab, wl = _lce_inputs(dev, rows=t_lce, rank=rank, world=world)
        hid.requires_grad_(True)
        wl.requires_grad_(True)
        group = dist.group.WORLD if world > 1 else None

        def lce():
            hid.grad = wl.grad = None
            fused_linear_cross_entropy(hid, wl, lab, vocab_parallel_group=group, vocab_start=rank * vloc,
                                       vocab_size=151936, **({"chunk_size": lce_chunk} if lce_chunk else {})).backward()

        def timed_whole(fn, n):  # collectives sit between the kernels: time the whole call, max over ranks
            ts = []
            for _ in range(n):
                flush.sum()
                dist.barrier()
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                torch.cuda.synchronize()
                t = torch.tensor([a.elapsed_time(b)], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ts.append(float(t))
            ts.sort()
            return ts[len(ts) // 2]

        if world == 1:
            ms = _kernel_ms(lce, flush, iters or 5, 2)
        else:
            for _ in range(2):
                lce()
            ms = timed_whole(lce, iters or 5)
        res = _tensor(ms, 61.1775e12 * t_lce / 16384, peaks)
        if world > 1:
            # the two exchanges of the call, timed by themselves on buffers of the call's sizes
            chunk = 8192
            mine = torch.zeros(chunk, 3, device=dev)
            gathered = torch.empty(world, chunk, 3, device=dev)
            dxf = torch.zeros(16384, 4096, device=dev)

            def stats_gather():
                dist.all_gather_into_tensor(gathered.view(-1), mine.view(-1))

            def dx_reduce():
                dist.all_reduce(dxf)

            for f in (stats_gather, dx_reduce):
                for _ in range(2):
                    f()
            res = {"ms": ms, "TFLOPs_all_gpus": res["TFLOPs"], "TFLOPs_per_gpu": res["TFLOPs"] / world,
                   "frac_of_bf16_burst_per_gpu": res["frac_of_bf16_burst"] / world, "n_gpus": world,
                   "collectives_ms": {"stats_all_gather_per_chunk": timed_whole(stats_gather, 5),
                                      "chunks": 2, "dhidden_all_reduce_fp32": timed_whole(dx_reduce, 5)},
                   "sharding": f"vocabulary: {vloc} lm_head rows per rank; one all-gather of [rows,3] fp32 statistics per "
                               "chunk, one fp32 all-reduce of d(hidden)", "algorithmic_TFLOP": 61.1775}
            del mine, gathered, dxf
        out[f"fused_linear_ce_{t_lce}x4096x151936_fwd_bwd"] = res
        del hid, lab, wl
    return out


def vp_parity_check(dev, rank, world):
    """Vocabulary-parallel fused loss over NCCL against the unsharded op on the same inputs
    (16384 x 4096 x 151936, config 3), both with all rows on every rank and with the rows sharded
    over the ranks.  Returns max-over-ranks errors; `ok` is False beyond loss 1e-3 / gradients 2e-2
    (relative to the largest reference magnitude)."""
    import torch
    import torch.distributed as dist

    from bastile_b200.ops.fused_linear_cross_entropy import fused_linear_cross_entropy

    vocab, rows = 151936, 16384
    vloc = vocab // world
    hid, lab, w_full = _lce_inputs(dev, full_weight=True)
    x0 = hid.clone().requires_grad_(True)
    w0 = w_full.clone().requires_grad_(True)
    loss0 = fused_linear_cross_entropy(x0, w0, lab)
    loss0.backward()
    dx_ref, dw_ref = x0.grad.float(), w0.grad[rank * vloc:(rank + 1) * vloc].float()
    sx, sw = float(dx_ref.abs().max()), float(w0.grad.float().abs().max())
    del w0, x0
    out = {}
    for shard_tokens in (False, True):
        xs = hid if not shard_tokens else hid[rank * (rows // world):(rank + 1) * (rows // world)]
        ls = lab if not shard_tokens else lab[rank * (rows // world):(rank + 1) * (rows // world)]
        x1 = xs.clone().requires_grad_(True)
        w1 = w_full[rank * vloc:(rank + 1) * vloc].clone().requires_grad_(True)
        loss1 = fused_linear_cross_entropy(x1, w1, ls, vocab_parallel_group=dist.group.WORLD, vocab_start=rank * vloc,
                                           shard_tokens=shard_tokens, vocab_size=vocab)
        loss1.backward()
        ref_rows = dx_ref if not shard_tokens else dx_ref[rank * (rows // world):(rank + 1) * (rows // world)]
        errs = torch.stack([(loss1.float() - loss0.float()).abs() / loss0.float().abs(),
                            (x1.grad.float() - ref_rows).abs().max() / sx,
                            (w1.grad.float() - dw_ref).abs().max() / sw]).to(torch.float64)
        dist.all_reduce(errs, op=dist.ReduceOp.MAX)
        e = [float(v) for v in errs.tolist()]
        out["shard_tokens" if shard_tokens else "all_rows_on_every_rank"] = {
            "loss_rel_err": e[0], "dx_max_abs_over_max": e[1], "dw_shard_max_abs_over_max": e[2]}
        del x1, w1
    checks = [v for v in out.values() if isinstance(v, dict)]
    out["ok"] = all(v["loss_rel_err"] <= 1e-3 and v["dx_max_abs_over_max"] <= 2e-2 and
                    v["dw_shard_max_abs_over_max"] <= 2e-2 for v in checks)
    out["loss_unsharded"] = float(loss0.detach())
    out["tolerance"] = {"loss": 1e-3, "gradients": 2e-2}
    return out


# ---------------------------------------------------------------------- one training run
class _LigerPatches:
    """apply_liger_kernel_to_qwen3 replaces attributes of transformers' qwen3 module for good;
    this puts them back afterwards."""

    NAMES = ("apply_rotary_pos_emb", "Qwen3RMSNorm", "Qwen3MLP")

    def __enter__(self):
        import transformers.models.qwen3.modeling_qwen3 as q3
        from liger_kernel.transformers import apply_liger_kernel_to_qwen3

        self.mod = q3
        self.saved = {n: getattr(q3, n) for n in self.NAMES}
        self.saved_fwd = q3.Qwen3ForCausalLM.forward
        # what the reference's benchmark applies (tests/benchmarks/e2e/qwen_8b_seqlen.py, phase "liger")
        apply_liger_kernel_to_qwen3(rope=True, rms_norm=True, swiglu=True, cross_entropy=False,
                                    fused_linear_cross_entropy=True)
        return self

    def __exit__(self, *exc):
        for n, v in self.saved.items():
            setattr(self.mod, n, v)
        self.mod.Qwen3ForCausalLM.forward = self.saved_fwd
        return False


def train_run(*, dev, rank, world, local, patches="bastile", parallel="single", optimizer="bastile", seq=SEQ_LEN,
              layers=36, intermediate=12288, steps=5, warmup=3, fused_layers=True, gemm_projections="acc",
              overlap_opt=True, tiles="auto", grad_checkpoint=False, measure_e2e=True, sample_clocks=False,
              master_weights=False, sweep=(), bucket_mb=1024, last_bucket_mb=None):
    """Build the model under the given patches / parallel wrapper / optimizer, run `warmup` untimed
    and `steps` timed steps (and, optionally, the same loop fed from pinned host memory), then the
    `sweep` entries (dicts with seq, steps, warmup, grad_checkpoint) on the same model.  Everything
    is torn down before returning."""
    import contextlib

    import torch
    import torch.distributed as dist
    from transformers import Qwen3Config

    import bastile_b200
    from bastile_b200 import _lib

    res = {"patches": patches, "parallel": parallel, "optimizer": optimizer}
    stack = contextlib.ExitStack()
    dynamic_tiles = tiles == "dynamic" or (tiles == "auto" and world > 1)
    applied = []
    if patches == "bastile":
        _lib.get_lib().bt_set_gemm_dynamic_tiles(1 if dynamic_tiles else 0)
        applied = bastile_b200.apply(fused_layers=fused_layers, gemm_projections=gemm_projections)
        expected = ["rms_norm_qwen3", "rope_qwen3", "swiglu_qwen3"]
        expected += ["decoder_layer_qwen3", "attention_qwen3"] if fused_layers else []
        assert applied == expected + ["fused_linear_cross_entropy"], applied
    else:
        bastile_b200.reset()
        if patches == "liger":
            stack.enter_context(_LigerPatches())
            applied = ["liger_kernel rope, rms_norm, swiglu, fused_linear_cross_entropy"]
    res["applied"] = applied
    import transformers.models.qwen3.modeling_qwen3 as q3

    cfg = Qwen3Config(**{**QWEN3_8B, "num_hidden_layers": layers, "intermediate_size": intermediate})
    cfg._attn_implementation = "sdpa"
    torch.manual_seed(1234)  # same initial weights on every rank
    prev = torch.get_default_dtype()
    # under FSDP "fp32 master" means fp32 shards that FSDP casts to bf16 for every layer's compute
    fsdp_fp32 = master_weights and world > 1 and parallel in ("fsdp", "fsdp-vp")
    torch.set_default_dtype(torch.float32 if fsdp_fp32 else torch.bfloat16)
    with torch.device(dev):
        model = q3.Qwen3ForCausalLM(cfg)
    torch.set_default_dtype(prev)
    model.train()
    if patches == "bastile" and fused_layers and gemm_projections == "qkv":
        from bastile_b200.ops.fused_layers import stack_qkv_weights

        res["qkv_blocks_stacked"] = stack_qkv_weights(model)
    ckpt_kwargs = {"gradient_checkpointing_kwargs": {"use_reentrant": False}}
    if grad_checkpoint:
        model.gradient_checkpointing_enable(**ckpt_kwargs)
    net = model
    parallelism = "single GPU"
    vp_on = False
    if world > 1 and parallel in ("fsdp", "fsdp-vp"):
        import functools

        from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
        from torch.distributed.fsdp import MixedPrecision, ShardingStrategy
        from torch.distributed.fsdp.wrap import transformer_auto_wrap_policy

        ignored = None
        if parallel == "fsdp-vp":
            # this rank keeps rows [rank*V/n, (rank+1)*V/n) of lm_head as an ordinary local parameter
            from bastile_b200.ops.fused_linear_cross_entropy import set_vocab_parallel

            vloc = cfg.vocab_size // world
            shard = model.lm_head.weight.data[rank * vloc:(rank + 1) * vloc].clone()
            model.lm_head.weight = torch.nn.Parameter(shard)
            set_vocab_parallel(dist.group.WORLD, vocab_start=rank * vloc, grad_hidden_scale=float(world),
                               vocab_size=cfg.vocab_size)
            vp_on = True
            ignored = [model.lm_head]
        mp = MixedPrecision(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16, buffer_dtype=torch.bfloat16)
        net = FSDP(model, sharding_strategy=ShardingStrategy.FULL_SHARD, mixed_precision=mp,
                   auto_wrap_policy=functools.partial(transformer_auto_wrap_policy,
                                                      transformer_layer_cls={q3.Qwen3DecoderLayer}),
                   use_orig_params=True, device_id=dev, ignored_modules=ignored)
        parallelism = (f"fsdp{world} FULL_SHARD, bf16 compute" + (" over fp32 parameter shards" if fsdp_fp32 else "") +
                       ", per-layer wrap" + (", lm_head vocabulary-parallel" if vp_on else ""))
    elif world > 1 and parallel == "ddp":
        from torch.nn.parallel import DistributedDataParallel as DDP

        net = DDP(model, device_ids=[local], gradient_as_bucket_view=True, bucket_cap_mb=256)
        parallelism = f"dp{world} (DistributedDataParallel, NCCL all-reduce, AdamW after the backward pass)"
    elif world > 1 and parallel == "sharded":
        parallelism = (f"dp{world} (bastile_b200.optim.ShardedAdamW: per-bucket NCCL reduce-scatter, AdamW on 1/{world} "
                       "of each bucket, all-gather of the parameters, all underneath the backward pass)")
    elif world > 1:
        raise SystemExit(f"--parallel {parallel} is not a multi-GPU mode")

    overlap = optimizer == "bastile" and world == 1 and overlap_opt
    if optimizer == "bastile" and world > 1 and parallel == "sharded":
        from bastile_b200.optim import ShardedAdamW

        opt = ShardedAdamW(net.parameters(), lr=1e-4, group=dist.group.WORLD, master_weights=master_weights,
                           bucket_mb=bucket_mb, last_bucket_mb=last_bucket_mb)
        opt_name = "bastile_b200.optim.ShardedAdamW" + (", fp32 master weights" if master_weights else
                                                        ", bf16 params and state")
    elif optimizer == "bastile":
        from bastile_b200.optim import AdamW

        # one process: every large parameter is updated as soon as its gradient is complete, on a side
        # stream underneath the rest of the backward pass (under DDP / FSDP gradients are only final after
        # the reduction, so the update stays in step())
        opt = AdamW(net.parameters(), lr=1e-4, overlap_backward=overlap,
                    master_weights=master_weights and not fsdp_fp32)
        opt_name = ("bastile_b200.optim.AdamW" + (", updates overlapped with the backward pass" if overlap else "") +
                    (", fp32 parameter shards and state (bf16 copies made by FSDP)" if fsdp_fp32 else
                     ", fp32 master weights" if master_weights else ", bf16 params and state"))
    else:
        if parallel == "sharded" and world > 1:
            raise SystemExit("--parallel sharded needs --optimizer bastile")
        opt = torch.optim.AdamW(net.parameters(), lr=1e-4, fused=True)
        opt_name = "torch.optim.AdamW(fused=True), bf16 params and state"
    res.update(parallelism=parallelism, optimizer_name=opt_name, gemm_tiles="dynamic" if dynamic_tiles else "fixed")

    torch.manual_seed(4321 + rank)  # different tokens per rank
    n_bufs = 4
    tail_events = []

    def step(ids, record_tail=False):
        opt.zero_grad(set_to_none=True)
        loss = net(input_ids=ids, labels=ids).loss
        loss.backward()
        if record_tail:
            a = torch.cuda.Event(enable_timing=True)
            a.record()
        opt.step()
        if record_tail:
            b = torch.cuda.Event(enable_timing=True)
            b.record()
            tail_events.append((a, b))
        return loss

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def measure(seq_len, n_steps, n_warm, e2e, clocks_on, record_ops):
        host_ids = [torch.randint(0, cfg.vocab_size, (1, seq_len)).pin_memory() for _ in range(n_bufs)]
        dev_ids = [h.to(dev) for h in host_ids]
        ids_in = torch.empty((1, seq_len), dtype=torch.int64, device=dev)
        out = {"seq": seq_len, "steps": n_steps, "warmup": n_warm}
        first = []
        for i in range(n_warm):
            ids_in.copy_(host_ids[i % n_bufs], non_blocking=True)
            first.append(float(step(ids_in).item()))
        out["first_losses"] = first
        if patches == "bastile":
            _lib.check_status(dev, "warm-up steps")
        torch.cuda.reset_peak_memory_stats()
        # ---- device-resident loop: `value`
        if record_ops:
            _lib.instr.reset(enabled=True)
        tail_events.clear()
        with (ClockSampler(local) if clocks_on else contextlib.nullcontext()) as clocks:
            fence()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(n_steps):
                loss = step(dev_ids[i % n_bufs], record_tail=True)
            e1.record()
            fence()
            ms_value = e0.elapsed_time(e1)
        if record_ops:
            out["launches"] = _lib.instr.launches
            out["op_ms"] = _lib.instr.elapsed_ms()
            _lib.instr.reset(enabled=False)
        out["tail_ms"] = sum(a.elapsed_time(b) for a, b in tail_events) / max(1, len(tail_events))
        out["last_loss"] = float(loss.item())
        if clocks_on:
            out["clocks"] = clocks.summary()
        ms_e2e = 0.0
        if e2e:
            # ---- end-to-end loop: pinned host ids -> device every step, loss read back every step
            fence()
            e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e2.record()
            for i in range(n_steps):
                ids_in.copy_(host_ids[i % n_bufs], non_blocking=True)
                step(ids_in).item()
            e3.record()
            fence()
            ms_e2e = e2.elapsed_time(e3)
        if patches == "bastile":
            _lib.check_all_status()
        t = torch.tensor([ms_value, ms_e2e, out["tail_ms"]], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_value, ms_e2e, out["tail_ms"] = (float(v) for v in t.tolist())
        tokens = seq_len * world * n_steps
        out.update(ms_value=ms_value, ms_per_step=ms_value / n_steps, tokens_per_s=tokens / (ms_value / 1e3),
                   peak_mem_GB=torch.cuda.max_memory_allocated() / 1e9)
        if e2e:
            out.update(ms_e2e=ms_e2e, e2e_tokens_per_s=tokens / (ms_e2e / 1e3), e2e_ms_per_step=ms_e2e / n_steps)
        return out

    try:
        res["main"] = measure(seq, steps, warmup, measure_e2e, sample_clocks, patches == "bastile")
        res["sweep"] = []
        for entry in sweep:
            try:
                if entry.get("grad_checkpoint") and not grad_checkpoint:
                    model.gradient_checkpointing_enable(**ckpt_kwargs)
                    grad_checkpoint = True
                r = measure(entry["seq"], entry.get("steps", 3), entry.get("warmup", 2), False, False, False)
                r["activation_checkpointing"] = bool(grad_checkpoint)
                res["sweep"].append(r)
            except torch.OutOfMemoryError as exc:
                res["sweep"].append({"seq": entry["seq"], "skipped": f"out of memory: {str(exc)[:80]}"})
                torch.cuda.empty_cache()
    finally:
        if vp_on:
            from bastile_b200.ops.fused_linear_cross_entropy import set_vocab_parallel

            set_vocab_parallel(None)
        if hasattr(opt, "close"):
            opt.close()  # gradient hooks keep model and optimizer alive otherwise
        del net, model, opt
        stack.close()
        gc.collect()
        torch.cuda.empty_cache()
    return res


def _slim(m):
    """The fields of a measure() result worth printing for a secondary run."""
    keep = ("seq", "steps", "warmup", "tokens_per_s", "ms_per_step", "peak_mem_GB", "tail_ms", "first_losses",
            "activation_checkpointing", "skipped")
    return {k: m[k] for k in keep if k in m}


def _row_ops_in_step(op_ms, steps, seq, layers, fused_layers, grad_checkpoint, hbm_gbs):
    """GB/s of the bandwidth-bound ops INSIDE the training step: algorithmic bytes of the calls a step makes over the
    CUDA-event time of those calls (the events `op_ms_per_step` is built from).  Only for the layout whose call
    list is known here: fused layers, no recomputation, Qwen3-8B heads (32 q + 8 k/v heads of 128)."""
    if not fused_layers or grad_checkpoint:
        return None
    h, hq, hk, d, e = QWEN3_8B["hidden_size"], 32, 8, 128, 2
    act = seq * h * e                                   # one [seq, hidden] bf16 tensor
    heads = seq * (hq + hk) * d * e                     # q and k of one layer
    cs = 2 * seq * d * e                                # cos and sin
    want = {  # name -> (calls per step, algorithmic bytes per step)
        "rmsnorm_fwd": (2 * layers + 1, layers * (2 * act + 4 * act) + 2 * act),       # norm; add + norm (x, r -> y, stream)
        "rmsnorm_bwd": (2 * layers + 1, 2 * layers * 4 * act + 3 * act),               # dy, x, d(stream) -> dx
        "rope_fwd": (layers, layers * (2 * heads + cs)),                               # q/k-norm + RoPE, q and k at once
        "rope_bwd": (layers, layers * (3 * heads + cs)),                               # d(out), heads -> d(heads)
    }
    out = {}
    for name, (calls, nbytes) in want.items():
        got = op_ms.get(name)
        if not got or got[0] != calls * steps or got[1] <= 0:
            continue
        ms = got[1] / steps
        gbs = nbytes / (ms / 1e3) / 1e9
        out[name] = {"calls_per_step": calls, "ms_per_step": ms, "algorithmic_GB_per_step": nbytes / 1e9,
                     "GBps": gbs, "frac_of_hbm_peak": gbs / hbm_gbs}
    if out:
        out["note"] = ("inside the step these kernels run at the power-capped clock (see clocks) and share HBM with the "
                       "AdamW updates of the side stream; per_op holds the same kernels timed alone")
    return out or None


def _traffic_from_profile():
    """DRAM bytes per launch of the dominant kernel, from the committed summary of its ncu capture."""
    p = ROOT / "profiles" / "gemm_kernel_pair_mlp_8192x4096x12288.json"
    try:
        d = json.loads(p.read_text())
        return float(d["dram_bytes_per_launch_mean"]), {"from_profile": True, "file": f"profiles/{p.name}",
                                                        "capture": d.get("command"), "note": d.get("note")}
    except Exception as exc:
        return None, {"from_profile": False, "error": repr(exc)}


# -------------------------------------------------------------------------- main arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seq", type=int, default=SEQ_LEN)
    ap.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"])
    ap.add_argument("--intermediate", type=int, default=QWEN3_8B["intermediate_size"],
                    help="MLP width (the reference's chart used 14336; Qwen3-8B itself has 12288)")
    ap.add_argument("--parallel", default="auto", choices=["auto", "sharded", "ddp", "fsdp", "fsdp-vp"],
                    help="N > 1: how the ranks cooperate (see the module docstring); auto = sharded")
    ap.add_argument("--fsdp", action="store_true", help="same as --parallel fsdp")
    ap.add_argument("--vocab-parallel", action="store_true", help="with --fsdp: same as --parallel fsdp-vp")
    ap.add_argument("--master-weights", action="store_true",
                    help="fp32 master parameters and moments in the bastile optimizers (bf16 parameters / fp32 master)")
    ap.add_argument("--grad-checkpoint", action="store_true",
                    help="recompute each decoder layer in the backward (needed for seq 32768 per rank: the saved "
                         "activations of 36 layers alone would exceed 180 GB)")
    ap.add_argument("--optimizer", default="bastile", choices=["bastile", "torch"],
                    help="bastile: bastile_b200.optim (streaming AdamW kernels); torch: "
                         "torch.optim.AdamW(fused=True), what the reference's benchmark loop uses")
    ap.add_argument("--no-fused-layers", action="store_true",
                    help="leave Qwen3DecoderLayer.forward / Qwen3Attention.forward as HF has them (by default the "
                         "bench applies bastile_b200.apply(fused_layers=True): residual adds folded into the norm "
                         "and down-projection kernels, q/k-norm + RoPE as one kernel)")
    ap.add_argument("--gemm-projections", default="acc", choices=["off", "acc", "dx", "all", "qkv"],
                    help="with fused layers: off = q/k/v/o_proj stay on nn.Linear (cuBLAS); acc = the same library "
                         "GEMMs, the q/k/v input gradient accumulated by the GEMMs (beta = 1) instead of added "
                         "afterwards; dx = their shared input "
                         "gradient from two bt_gemm_ex launches; all = every product of theirs on bt_gemm_ex; qkv = "
                         "q/k/v weights stacked in memory and the three projections run as one product each way")
    ap.add_argument("--no-overlap-optimizer", action="store_true",
                    help="single GPU: run the whole AdamW step after the backward pass instead of updating each "
                         "large parameter underneath it as soon as its gradient is complete")
    ap.add_argument("--tiles", default="auto", choices=["auto", "fixed", "dynamic"],
                    help="how the GEMM's CTA pairs get their tiles: dealt round-robin at launch (fixed) or drawn from "
                         "a global counter at run time (dynamic: bt_set_gemm_dynamic_tiles(1)); auto = dynamic when "
                         "NCCL collectives share the GPU with the backward pass (more than one rank), else fixed")
    ap.add_argument("--tile-stores", default="on", choices=["on", "off"],
                    help="16-bit GEMM results through shared memory + tile stores (on, the library's default) or "
                         "stored by each epilogue thread from registers (off: bt_set_gemm_tile_stores(0))")
    ap.add_argument("--bucket-mb", type=int, default=1024, help="--parallel sharded: size of a gradient bucket")
    ap.add_argument("--last-bucket-mb", type=int, default=None,
                    help="--parallel sharded: bucket size for the parameters whose gradients arrive last (default: a "
                         "quarter of --bucket-mb; equal to --bucket-mb = no tapering)")
    ap.add_argument("--group-rows", type=int, default=0,
                    help="tile rasterisation of the GEMMs: row tiles walked per column tile (0 = library default)")
    ap.add_argument("--dependent-launch", default="on", choices=["on", "off"],
                    help="launch the library's kernels as programmatic dependents of their predecessors (on, the "
                         "library's default) or the ordinary way (off: bt_set_dependent_launch(0))")
    ap.add_argument("--no-per-op", action="store_true")
    ap.add_argument("--only-op", default=None, choices=["rmsnorm", "rope", "swiglu", "adamw", "mlp", "lce"],
                    help="run just this op's forward+backward micro-benchmark (small case for profilers)")
    ap.add_argument("--op-iters", type=int, default=None)
    ap.add_argument("--lce-chunk", type=int, default=None, help="with --only-op lce: rows per chunk (chunk_size=)")
    ap.add_argument("--op-rows", type=int, default=None,
                    help="with --only-op mlp / lce: token rows instead of 8192 / 16384 (small case for a profiler)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the main timed loop: no sequence sweep, comparators, DDP / FSDP companion runs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the bastile_b200 ops have no CPU implementation")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from bastile_b200 import _lib

    peaks, peak_kind = load_peaks()
    _lib.get_lib().bt_set_gemm_tile_stores(1 if args.tile_stores == "on" else 0)
    _lib.get_lib().bt_set_gemm_group_rows(args.group_rows)
    _lib.get_lib().bt_set_dependent_launch(1 if args.dependent_launch == "on" else 0)
    if args.only_op:
        with ClockSampler(local) as op_clocks:
            res = per_op_bench(peaks, only=args.only_op, iters=args.op_iters, rows=args.op_rows, lce_chunk=args.lce_chunk)
        _lib.check_status(dev, "per-op benchmark")
        if rank == 0:
            print(json.dumps({"per_op": res, "peaks": peaks, "peak_kind": peak_kind, "n_gpus": world,
                              "clocks": op_clocks.summary()}), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    parallel = args.parallel
    if args.fsdp:
        parallel = "fsdp-vp" if args.vocab_parallel else "fsdp"
    if parallel == "auto":
        parallel = "sharded" if (world > 1 and args.optimizer == "bastile") else ("ddp" if world > 1 else "single")
    if world == 1:
        parallel = "single"
    fused_layers = not args.no_fused_layers
    grad_checkpoint = args.grad_checkpoint or args.seq >= 32768
    common = dict(dev=dev, rank=rank, world=world, local=local, layers=args.layers, fused_layers=fused_layers,
                  gemm_projections=args.gemm_projections, tiles=args.tiles)
    extras = not args.no_extras and args.layers == QWEN3_8B["num_hidden_layers"]

    sweep = []
    if extras and world == 1 and args.seq == SEQ_LEN and not grad_checkpoint:
        # the reference's chart runs 256 ... 32768 (tests/benchmarks/e2e/qwen_8b_seqlen.py:47): the short ones
        # show host time per step, the long ones the attention share
        sweep = [{"seq": 256, "steps": 5, "warmup": 3}, {"seq": 512, "steps": 5, "warmup": 3},
                 {"seq": 2048, "steps": 3, "warmup": 2}, {"seq": 4096, "steps": 3, "warmup": 2},
                 {"seq": 16384, "steps": 3, "warmup": 2}]
    main_run = train_run(**common, patches="bastile", parallel=parallel, optimizer=args.optimizer, seq=args.seq,
                         intermediate=args.intermediate, steps=args.steps, warmup=args.warmup,
                         overlap_opt=not args.no_overlap_optimizer, grad_checkpoint=grad_checkpoint,
                         measure_e2e=True, sample_clocks=True, master_weights=args.master_weights, sweep=sweep,
                         bucket_mb=args.bucket_mb, last_bucket_mb=args.last_bucket_mb)
    m = main_run["main"]
    op_ms = m["op_ms"]
    seq = args.seq

    # ---- roofline of the dominant kernel: the tcgen05 GEMM under the MLP block
    hdim, inter = QWEN3_8B["hidden_size"], args.intermediate
    mlp_calls, mlp_ms = 0, 0.0
    for name in ("mlp_fwd", "mlp_bwd"):
        c, t = op_ms.get(name, (0, 0.0))
        mlp_calls += c
        mlp_ms += t
    blocks = mlp_calls // 2
    if grad_checkpoint:  # every block's forward runs twice; events cover all of it, so do the flops
        blocks_flops = 12 * 2.0 * seq * hdim * inter * op_ms.get("mlp_bwd", (0, 0))[0]
        gemm_launches = 2 * op_ms.get("mlp_fwd", (0, 0))[0] + 4 * op_ms.get("mlp_bwd", (0, 0))[0]
    else:
        blocks_flops = 9 * 2.0 * seq * hdim * inter * blocks
        gemm_launches = 6 * blocks
    achieved = blocks_flops / (mlp_ms / 1e3) / 1e12 if mlp_ms > 0 else None
    peak_tf = peaks["bf16_tflops_sustained"]
    traffic, traffic_src = _traffic_from_profile()
    roofline = {"bound": "tensor", "kernel": "bt::gemm::gemm_kernel_pair, tcgen05 cta_group::2 (6 launches per MLP block: gate|up fused, "
                                             "down (+ residual), dh->dgate/dup, dWd, dWg|dWu stacked, dx)",
                "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf if achieved else None,
                "peak_kind": f"{peak_kind} cuBLAS bf16, sustained (kernel timed inside a long step); burst {peaks['bf16_tflops']}",
                "frac_of_burst": achieved / peaks["bf16_tflops"] if achieved else None,
                "flops_per_launch": blocks_flops / gemm_launches if gemm_launches else None,
                "avg_launch_ms": mlp_ms / gemm_launches if gemm_launches else None, "launches_timed": gemm_launches,
                "traffic": traffic, "traffic_source": traffic_src}

    line = {"metric": METRIC, "value": m["tokens_per_s"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": m["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"qwen3-8b ({args.layers} layers, hidden 4096, intermediate {args.intermediate}, vocab 151936) seq {seq} "
                                   "batch 1 fwd+bwd+AdamW, random init",
                       "global_batch_tokens": seq * world, "seq_len": seq,
                       "parallelism": main_run["parallelism"],
                       "attention": "torch SDPA", "activation_checkpointing": bool(grad_checkpoint),
                       "gemm_tiles": main_run["gemm_tiles"], "fused_layers": fused_layers,
                       "gemm_projections": args.gemm_projections if fused_layers else "off",
                       "optimizer": main_run["optimizer_name"],
                       "l2": "each step streams ~65 GB of weights, gradients and optimizer state: far larger than the 126 MB L2"},
            "e2e": {"value": m["e2e_tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": seq * 8,
                    "d2h_bytes_per_step": 4, "ms_per_step": m["e2e_ms_per_step"]},
            "gpu_launches": m["launches"], "clocks": m["clocks"], "roofline": roofline, "loss": m["last_loss"],
            "op_ms_per_step": {k: v[1] / args.steps for k, v in op_ms.items()},
            "optimizer_tail_ms_per_step": m["tail_ms"],
            "optimizer_tail_note": "device time from the end of the backward pass on the main stream to the end of "
                                   "optimizer.step(): what the optimizer and (N > 1) the gradient / parameter "
                                   "collectives leave exposed",
            "peak_mem_GB": m["peak_mem_GB"], "applied": main_run["applied"]}
    if main_run["sweep"]:
        line["seq_sweep"] = [_slim(r) for r in main_run["sweep"]]
    row_ops = _row_ops_in_step(op_ms, args.steps, seq, args.layers, fused_layers, grad_checkpoint, peaks["hbm_gbs"])
    if row_ops:
        line["row_ops_in_step"] = row_ops
    rc = 0

    def guarded(name, fn):
        """A companion measurement must not void the headline: record its failure instead."""
        try:
            return fn()
        except Exception as exc:  # noqa: BLE001
            failure = {"skipped": f"{type(exc).__name__}: {str(exc)[:200]}", "what": name}
        # the exception (and the frames its traceback held) is gone here: now memory can be returned
        gc.collect()
        torch.cuda.empty_cache()
        return failure

    if world == 1:
        line["reference_published"] = REFERENCE_CHART
        if not args.no_per_op:
            with ClockSampler(local) as op_clocks:
                line["per_op"] = guarded("per_op", lambda: per_op_bench(peaks))
            # the micro-benchmarks leave the GPU idle between calls, so the median says little; the
            # highest clock seen tells a box whose clocks are held down from a healthy one
            line["per_op_clocks"] = op_clocks.summary()
            torch.cuda.empty_cache()
        if extras and seq == SEQ_LEN:
            sw = guarded("intermediate 14336", lambda: train_run(
                **common, patches="bastile", parallel="single", optimizer=args.optimizer, seq=seq, intermediate=14336,
                steps=3, warmup=3, measure_e2e=False))
            line.setdefault("seq_sweep", []).append(
                {"intermediate": 14336, "note": "the reference chart's MLP width (12.0 K tokens/s on its stack)",
                 **(_slim(sw["main"]) if "main" in sw else sw)})
            comps = {}
            for name, kw in (("hf_eager_cuda", dict(patches="eager", optimizer="torch")),
                             ("liger", dict(patches="liger", optimizer="torch"))):
                r = guarded(name, lambda kw=kw: train_run(**common, parallel="single", seq=seq,
                                                          intermediate=args.intermediate, steps=3, warmup=3,
                                                          measure_e2e=False, **kw))
                if "main" in r:
                    comps[name] = {**_slim(r["main"]), "optimizer": r["optimizer_name"], "applied": r["applied"]}
                    comps["x_over_" + name.replace("hf_eager_cuda", "eager")] = m["tokens_per_s"] / r["main"]["tokens_per_s"]
                else:
                    comps[name] = r
            comps["note"] = ("same GPU, same loop, same model shape and torch; hf_eager_cuda is what reset() restores; "
                             "liger = liger_kernel's qwen3 patches as the reference's benchmark applies them. The "
                             "reference's chart has bastile/pytorch = 1.24 and bastile/liger = 1.165 at seq 8192.")
            line["comparators"] = comps
        if not args.no_cpu_baseline:
            v, times, threads = cpu_reference_sample(256)
            line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "reference",
                                    "sample": "HF transformers eager Qwen3 (unpatched), fp32, Qwen3-8B shapes at 256 tokens: "
                                              "36 x (decoder layer fwd+bwd) + (final norm + lm_head + cross-entropy fwd+bwd) "
                                              "+ AdamW scaled to 8.19 B parameters; "
                                              + json.dumps({k: round(v, 3) for k, v in times.items()})}
    else:
        if not args.no_per_op:
            line["per_op"] = guarded("per_op lce", lambda: per_op_bench(peaks, only="lce"))
            vp = guarded("vp_parity", lambda: vp_parity_check(dev, rank, world))
            line["vp_parity"] = vp
            if vp.get("ok") is False:
                rc = 3
            torch.cuda.empty_cache()
        if extras and seq == SEQ_LEN:
            if parallel != "ddp":
                d = guarded("ddp", lambda: train_run(**common, patches="bastile", parallel="ddp",
                                                     optimizer=args.optimizer, seq=seq, intermediate=args.intermediate,
                                                     steps=3, warmup=args.warmup, measure_e2e=False))
                if "main" in d:
                    mine, theirs = m["first_losses"], d["main"]["first_losses"]
                    rel = max(abs(a - b) / abs(b) for a, b in zip(mine, theirs))
                    line["ddp"] = {**_slim(d["main"]), "parallelism": d["parallelism"],
                                   "first_losses_main": mine, "loss_rel_diff_vs_main": rel, "tolerance": 2e-3}
                    if rel > 2e-3:
                        rc = rc or 4
                else:
                    line["ddp"] = d
            f = guarded("fsdp-vp", lambda: train_run(
                **common, patches="bastile", parallel="fsdp-vp", optimizer=args.optimizer, seq=seq,
                intermediate=args.intermediate, steps=3, warmup=3, measure_e2e=False,
                sweep=[{"seq": 32768, "steps": 2, "warmup": 2, "grad_checkpoint": True}]))
            fm = guarded("fsdp-vp, fp32 master", lambda: train_run(
                **common, patches="bastile", parallel="fsdp-vp", optimizer=args.optimizer, seq=32768,
                intermediate=args.intermediate, steps=2, warmup=2, measure_e2e=False, grad_checkpoint=True,
                master_weights=True))
            if "main" in f:
                line["sharded"] = {"parallelism": f["parallelism"], "optimizer": f["optimizer_name"],
                                   "seq_8192_per_rank": _slim(f["main"]),
                                   "seq_32768_per_rank": [_slim(r) for r in f["sweep"]],
                                   "seq_32768_per_rank_fp32_master": (
                                       {**_slim(fm["main"]), "parallelism": fm["parallelism"],
                                        "optimizer": fm["optimizer_name"]} if "main" in fm else fm),
                                   "note": "FSDP FULL_SHARD per decoder layer (the reference's qwen_8b_fsdp.py recipe) with "
                                           "the lm_head rows sharded over the ranks and the fused loss vocabulary-parallel; "
                                           "32768 tokens per rank runs with activation checkpointing; tokens/s is the "
                                           "whole job's"}
            else:
                line["sharded"] = f
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rc:
        sys.exit(rc)


if __name__ == "__main__":
    main()
