#!/usr/bin/env python
"""Benchmark of the Qwen3 training hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is a full training step (forward, backward, AdamW step) of a random-init
Qwen3-8B-shaped model (36 layers, hidden 4096, 32/8 heads, head_dim 128,
intermediate 12288, vocab 151936, bf16) on one sequence of 8192 synthetic tokens,
with RMSNorm, RoPE, the SwiGLU MLP and the fused lm_head + cross-entropy running on
the bastile_b200 kernels and the optimizer step on bastile_b200.optim.AdamW (--optimizer torch
selects torch.optim.AdamW as in the reference's own benchmark,
tests/benchmarks/e2e/qwen_8b_seqlen.py:80-203); attention and the q/k/v/o projections are
stock PyTorch.  By default the patch set is `apply(fused_layers=True)` (residual adds folded into
the norm / down-projection kernels, q/k-norm + RoPE as one kernel; --no-fused-layers for exactly
the reference's four patches) and, on one GPU, the optimizer updates each large parameter
underneath the backward pass as soon as its gradient is complete (--no-overlap-optimizer).
With N > 1 (launched by torchrun,
one rank per GPU) every rank steps its own sequence and gradients are averaged by
DistributedDataParallel over NCCL: weak scaling by tokens; the GEMM then draws its tiles at
run time (--tiles) because NCCL kernels share the SMs with the backward pass.

Rank 0 prints ONE JSON line.  `value` is tokens/s with the step's inputs already on
the device; `e2e` is the same loop fed from pinned host buffers with the loss read
back every step.  `roofline` describes the dominant kernel (the tcgen05 GEMM that
runs the MLP block) from CUDA events recorded around its launches inside the timed
steps.  `per_op` holds the forward+backward micro-benchmarks of the four ops at the
per-op benchmark shapes.  `cpu_baseline` (N = 1 only) times HF eager on the host cores on a
bounded sample.  `--impl reference` prints that CPU measurement as its own line.
"""

from __future__ import annotations

import argparse
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
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


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
    vals = []
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_reference_sample(seq)
    t_begin = time.perf_counter()
    for _ in range(max(1, args.steps)):
        v, times, threads = cpu_reference_sample(seq)
        vals.append(v)
        if time.perf_counter() - t_begin > 240:  # stay within a few minutes whatever K is
            break
    vals.sort()
    value = vals[len(vals) // 2]
    sample = (f"HF transformers eager Qwen3 (what bastile.reset() restores), fp32, Qwen3-8B shapes at {seq} tokens: "
              f"36 x (decoder layer fwd+bwd) + (final norm + lm_head + cross-entropy fwd+bwd) + AdamW scaled to 8.19 B "
              f"parameters; median of {len(vals)} samples; last: {json.dumps({k: round(v, 3) for k, v in times.items()})}")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": len(vals), "warmup": min(args.warmup, 1), "ms_per_step": SEQ_LEN / value * 1e3,
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


def per_op_bench(peaks, only=None, iters=None):
    """Forward+backward of each op at the per-op benchmark shapes (bf16, seed 1), called through
    the public ops; the time is that of the kernels (events around the library calls)."""
    import torch

    from bastile_b200.ops.fused_linear_cross_entropy import fused_linear_cross_entropy
    from bastile_b200.ops.rms_norm import rms_norm
    from bastile_b200.ops.rope import RoPEFunction
    from bastile_b200.ops.swiglu import SwiGLUMLPFunction

    dev = "cuda"
    torch.manual_seed(1)
    flush = torch.zeros(64 << 20, dtype=torch.int32, device=dev)  # 256 MiB
    out = {}
    bf = torch.bfloat16
    want = lambda name: only is None or only == name  # noqa: E731

    if want("rmsnorm"):
        for m, n in ((8192, 4096), (262144, 128)):
            x = torch.randn(m, n, device=dev, dtype=bf).requires_grad_(True)
            w = (1 + 0.02 * torch.randn(n, device=dev)).to(bf).requires_grad_(True)
            dy = torch.randn(m, n, device=dev, dtype=bf)

            def rms():
                x.grad = w.grad = None
                rms_norm(x, w, 1e-6).backward(dy)

            byts = 5 * m * n * 2 + 8 * m + 6 * n
            out[f"rmsnorm_{m}x{n}_fwd_bwd"] = _hbm(_kernel_ms(rms, flush, iters or 20, 5), byts, peaks)
            del x, w, dy

    if want("rmsnorm"):
        from bastile_b200.ops.fused_layers import add_rms_norm

        m, n = 8192, 4096
        x = torch.randn(m, n, device=dev, dtype=bf).requires_grad_(True)
        r = torch.randn(m, n, device=dev, dtype=bf)
        w = (1 + 0.02 * torch.randn(n, device=dev)).to(bf).requires_grad_(True)
        dy, ds = torch.randn(m, n, device=dev, dtype=bf), torch.randn(m, n, device=dev, dtype=bf)

        def add_rms():
            x.grad = w.grad = None
            y, stream = add_rms_norm(x, r, w, 1e-6)
            torch.autograd.backward([y, stream], [dy, ds])

        # fwd: x, residual in; sum, y out.  bwd: dy, sum, d(stream) in; dx out.
        byts = 8 * m * n * 2 + 8 * m + 6 * n
        out[f"add_rmsnorm_{m}x{n}_fwd_bwd"] = _hbm(_kernel_ms(add_rms, flush, iters or 20, 5), byts, peaks)
        del x, r, w, dy, ds

    if want("rope"):
        from bastile_b200.ops.fused_layers import qk_norm_rope as fused_qk

        inv = 1.0 / (1e6 ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128))
        emb = torch.outer(torch.arange(8192, dtype=torch.float32), inv)
        emb = torch.cat((emb, emb), -1)
        cos, sin = emb.cos()[None].to(dev, bf), emb.sin()[None].to(dev, bf)
        xq = torch.randn(1, 8192, 32, 128, device=dev, dtype=bf).requires_grad_(True)
        xk = torch.randn(1, 8192, 8, 128, device=dev, dtype=bf).requires_grad_(True)
        wq = torch.ones(128, device=dev, dtype=bf, requires_grad=True)
        wk = torch.ones(128, device=dev, dtype=bf, requires_grad=True)
        dq, dk = torch.randn_like(xq), torch.randn_like(xk)

        def qk_norm_rope():
            xq.grad = xk.grad = wq.grad = wk.grad = None
            qo, ko = fused_qk(xq, xk, wq, wk, cos, sin)
            torch.autograd.backward([qo, ko], [dq, dk])

        # fwd: heads in, heads out; bwd: d(out), heads in, d(heads) out; plus the cos/sin half rows
        byts = 5 * (xq.numel() + xk.numel()) * 2 + 2 * 2 * 8192 * 64 * 2
        out["qk_norm_rope_q32_k8_8192x128_fwd_bwd"] = _hbm(_kernel_ms(qk_norm_rope, flush, iters or 20, 5), byts, peaks)
        del xq, xk, dq, dk

    if want("rope"):
        q = torch.randn(1, 32, 8192, 128, device=dev, dtype=bf).requires_grad_(True)
        k = torch.randn(1, 8, 8192, 128, device=dev, dtype=bf).requires_grad_(True)
        inv = 1.0 / (1e6 ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128))
        emb = torch.outer(torch.arange(8192, dtype=torch.float32), inv)
        emb = torch.cat((emb, emb), -1)
        cos, sin = emb.cos()[None].to(dev, bf), emb.sin()[None].to(dev, bf)
        dq, dk = torch.randn_like(q), torch.randn_like(k)

        def rope():
            q.grad = k.grad = None
            qo, ko = RoPEFunction.apply(q * 1, k * 1, cos, sin)  # `* 1`: the op rotates its input in place
            torch.autograd.backward([qo, ko], [dq, dk])

        out["rope_q32_k8_8192x128_fwd_bwd"] = _hbm(_kernel_ms(rope, flush, iters or 20, 5), 339.74e6, peaks)
        del q, k, dq, dk

    if want("mlp"):
        xm = torch.randn(8192, 4096, device=dev, dtype=bf).requires_grad_(True)
        wg = (torch.randn(12288, 4096, device=dev) * 0.02).to(bf).requires_grad_(True)
        wu = (torch.randn(12288, 4096, device=dev) * 0.02).to(bf).requires_grad_(True)
        wd = (torch.randn(4096, 12288, device=dev) * 0.02).to(bf).requires_grad_(True)
        dym = torch.randn(8192, 4096, device=dev, dtype=bf)

        def mlp():
            xm.grad = wg.grad = wu.grad = wd.grad = None
            SwiGLUMLPFunction.apply(xm, wg, wu, wd).backward(dym)

        out["swiglu_mlp_8192x4096x12288_fwd_bwd"] = _tensor(_kernel_ms(mlp, flush, iters or 10, 3), 7.4217e12, peaks)
        del xm, wg, wu, wd, dym

    if want("lce"):
        import torch.distributed as dist

        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        vloc = 151936 // world  # 75968 / 37984 / 18992 rows of lm_head per rank at 2 / 4 / 8 GPUs
        gen = torch.Generator(device=dev).manual_seed(1)  # same hidden states and labels on every rank
        hid = torch.randn(16384, 4096, device=dev, dtype=bf, generator=gen).requires_grad_(True)
        lab = torch.randint(0, 151936, (16384,), device=dev, generator=gen)
        lab[torch.rand(16384, device=dev, generator=gen) < 0.05] = -100
        wl = (torch.randn(vloc, 4096, device=dev, dtype=bf) * 0.02).requires_grad_(True)
        group = dist.group.WORLD if world > 1 else None

        def lce():
            hid.grad = wl.grad = None
            fused_linear_cross_entropy(hid, wl, lab, vocab_parallel_group=group, vocab_start=rank * vloc).backward()

        if world == 1:
            ms = _kernel_ms(lce, flush, iters or 5, 2)
        else:  # collectives sit between the kernels: time the whole call, max over ranks
            for _ in range(2):
                lce()
            ts = []
            for _ in range(iters or 5):
                flush.sum()
                dist.barrier()
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                lce()
                b.record()
                torch.cuda.synchronize()
                t = torch.tensor([a.elapsed_time(b)], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ts.append(float(t))
            ts.sort()
            ms = ts[len(ts) // 2]
        res = _tensor(ms, 61.1775e12, peaks)
        if world > 1:
            res = {"ms": ms, "TFLOPs_all_gpus": res["TFLOPs"], "TFLOPs_per_gpu": res["TFLOPs"] / world,
                   "frac_of_bf16_burst_per_gpu": res["frac_of_bf16_burst"] / world, "n_gpus": world,
                   "sharding": f"vocabulary: {vloc} lm_head rows per rank; one all-gather of [rows,3] fp32 statistics per "
                               "chunk, one fp32 all-reduce of d(hidden)", "algorithmic_TFLOP": 61.1775}
        out["fused_linear_ce_16384x4096x151936_fwd_bwd"] = res
    return out


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
    ap.add_argument("--fsdp", action="store_true",
                    help="N > 1: FullyShardedDataParallel FULL_SHARD with bf16 mixed precision, wrapped per decoder layer "
                         "(the reference's tests/benchmarks/e2e/qwen_8b_fsdp.py:161-168) instead of DDP")
    ap.add_argument("--vocab-parallel", action="store_true",
                    help="with --fsdp: lm_head rows sharded over ranks and the fused loss run vocabulary-parallel")
    ap.add_argument("--grad-checkpoint", action="store_true",
                    help="recompute each decoder layer in the backward (needed for seq 32768 per rank: the saved "
                         "activations of 36 layers alone would exceed 180 GB)")
    ap.add_argument("--optimizer", default="bastile", choices=["bastile", "torch"],
                    help="bastile: bastile_b200.optim.AdamW (one streaming kernel per tensor); torch: "
                         "torch.optim.AdamW(fused=True), what the reference's benchmark loop uses")
    ap.add_argument("--no-fused-layers", action="store_true",
                    help="leave Qwen3DecoderLayer.forward / Qwen3Attention.forward as HF has them (by default the "
                         "bench applies bastile_b200.apply(fused_layers=True): residual adds folded into the norm "
                         "and down-projection kernels, q/k-norm + RoPE as one kernel)")
    ap.add_argument("--gemm-projections", default="off", choices=["off", "dx", "all"],
                    help="with fused layers: off = q/k/v/o_proj stay on nn.Linear (cuBLAS); dx = their shared input "
                         "gradient from two bt_gemm_ex launches; all = every product of theirs on bt_gemm_ex")
    ap.add_argument("--no-overlap-optimizer", action="store_true",
                    help="single GPU: run the whole AdamW step after the backward pass instead of updating each "
                         "large parameter underneath it as soon as its gradient is complete")
    ap.add_argument("--tiles", default="auto", choices=["auto", "fixed", "dynamic"],
                    help="how the GEMM's CTA pairs get their tiles: dealt round-robin at launch (fixed) or drawn from "
                         "a global counter at run time (dynamic: bt_set_gemm_dynamic_tiles(1)); auto = dynamic when "
                         "NCCL collectives share the GPU with the backward pass (more than one rank), else fixed")
    ap.add_argument("--no-per-op", action="store_true")
    ap.add_argument("--only-op", default=None, choices=["rmsnorm", "rope", "mlp", "lce"],
                    help="run just this op's forward+backward micro-benchmark (small case for profilers)")
    ap.add_argument("--op-iters", type=int, default=None)
    ap.add_argument("--no-cpu-baseline", action="store_true")
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

    import bastile_b200
    from bastile_b200 import _lib
    from transformers import Qwen3Config, Qwen3ForCausalLM

    if args.only_op:
        peaks, peak_kind = load_peaks()
        res = per_op_bench(peaks, only=args.only_op, iters=args.op_iters)
        _lib.check_status(dev, "per-op benchmark")
        if rank == 0:
            print(json.dumps({"per_op": res, "peaks": peaks, "peak_kind": peak_kind, "n_gpus": world}), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    fused_layers = not args.no_fused_layers
    dynamic_tiles = args.tiles == "dynamic" or (args.tiles == "auto" and world > 1)
    _lib.get_lib().bt_set_gemm_dynamic_tiles(1 if dynamic_tiles else 0)
    applied = bastile_b200.apply(fused_layers=fused_layers, gemm_projections=args.gemm_projections)
    expected = ["rms_norm_qwen3", "rope_qwen3", "swiglu_qwen3"]
    expected += ["decoder_layer_qwen3", "attention_qwen3"] if fused_layers else []
    assert applied == expected + ["fused_linear_cross_entropy"], applied
    peaks, peak_kind = load_peaks()

    cfg = Qwen3Config(**{**QWEN3_8B, "num_hidden_layers": args.layers, "intermediate_size": args.intermediate})
    cfg._attn_implementation = "sdpa"
    torch.manual_seed(1234)  # same initial weights on every rank
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(dev):
        model = Qwen3ForCausalLM(cfg)
    torch.set_default_dtype(prev)
    model.train()
    if args.grad_checkpoint or args.seq >= 32768:
        args.grad_checkpoint = True
        model.gradient_checkpointing_enable(gradient_checkpointing_kwargs={"use_reentrant": False})
    net = model
    parallelism = "single GPU"
    if world > 1 and args.fsdp:
        import functools

        from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
        from torch.distributed.fsdp import MixedPrecision, ShardingStrategy
        from torch.distributed.fsdp.wrap import transformer_auto_wrap_policy
        from transformers.models.qwen3.modeling_qwen3 import Qwen3DecoderLayer

        ignored = None
        if args.vocab_parallel:
            # this rank keeps rows [rank*V/n, (rank+1)*V/n) of lm_head as an ordinary local parameter
            from bastile_b200.ops.fused_linear_cross_entropy import set_vocab_parallel

            vloc = cfg.vocab_size // world
            shard = model.lm_head.weight.data[rank * vloc:(rank + 1) * vloc].clone()
            model.lm_head.weight = torch.nn.Parameter(shard)
            set_vocab_parallel(dist.group.WORLD, vocab_start=rank * vloc, grad_hidden_scale=float(world))
            ignored = [model.lm_head]
        mp = MixedPrecision(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16, buffer_dtype=torch.bfloat16)
        net = FSDP(model, sharding_strategy=ShardingStrategy.FULL_SHARD, mixed_precision=mp,
                   auto_wrap_policy=functools.partial(transformer_auto_wrap_policy,
                                                      transformer_layer_cls={Qwen3DecoderLayer}),
                   use_orig_params=True, device_id=dev, ignored_modules=ignored)
        parallelism = (f"fsdp{world} FULL_SHARD bf16, per-layer wrap" +
                       (", lm_head vocabulary-parallel" if args.vocab_parallel else ""))
    elif world > 1:
        from torch.nn.parallel import DistributedDataParallel as DDP

        net = DDP(model, device_ids=[local], gradient_as_bucket_view=True, bucket_cap_mb=256)
        parallelism = f"dp{world} (DistributedDataParallel, NCCL)"
    overlap_opt = args.optimizer == "bastile" and world == 1 and not args.no_overlap_optimizer
    if args.optimizer == "bastile":
        from bastile_b200.optim import AdamW

        # one process: every large parameter is updated as soon as its gradient is complete, on a side
        # stream underneath the rest of the backward pass (under DDP / FSDP gradients are only final after
        # the reduction, so the update stays in step())
        opt = AdamW(net.parameters(), lr=1e-4, overlap_backward=overlap_opt)
    else:
        opt = torch.optim.AdamW(net.parameters(), lr=1e-4, fused=True)

    torch.manual_seed(4321 + rank)  # different tokens per rank
    seq = args.seq
    n_bufs = 4
    host_ids = [torch.randint(0, cfg.vocab_size, (1, seq)).pin_memory() for _ in range(n_bufs)]
    dev_ids = [h.to(dev) for h in host_ids]
    ids_in = torch.empty((1, seq), dtype=torch.int64, device=dev)

    def step(ids):
        opt.zero_grad(set_to_none=True)
        loss = net(input_ids=ids, labels=ids).loss
        loss.backward()
        opt.step()
        return loss

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        ids_in.copy_(host_ids[i % n_bufs], non_blocking=True)
        step(ids_in).item()
    _lib.check_status(dev, "warm-up steps")

    # ---- device-resident loop: `value`
    _lib.instr.reset(enabled=True)
    with ClockSampler(local) as clocks:
        fence()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            loss = step(dev_ids[i % n_bufs])
        e1.record()
        fence()
        ms_value = e0.elapsed_time(e1)
    launches = _lib.instr.launches
    op_ms = _lib.instr.elapsed_ms()
    _lib.instr.reset(enabled=False)
    last_loss = float(loss.item())

    # ---- end-to-end loop: pinned host ids -> device every step, loss read back every step
    fence()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for i in range(args.steps):
        ids_in.copy_(host_ids[i % n_bufs], non_blocking=True)
        step(ids_in).item()
    e3.record()
    fence()
    ms_e2e = e2.elapsed_time(e3)
    _lib.check_all_status()

    t = torch.tensor([ms_value, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_value, ms_e2e = (float(v) for v in t.tolist())
    tokens = seq * world * args.steps
    value = tokens / (ms_value / 1e3)
    e2e_value = tokens / (ms_e2e / 1e3)

    # ---- roofline of the dominant kernel: the tcgen05 GEMM under the MLP block
    hdim, inter = cfg.hidden_size, cfg.intermediate_size
    mlp_calls, mlp_ms = 0, 0.0
    for name in ("mlp_fwd", "mlp_bwd"):
        c, m = op_ms.get(name, (0, 0.0))
        mlp_calls += c
        mlp_ms += m
    gemm_launches = 6 * (mlp_calls // 2) if mlp_calls else 0
    mlp_flops = 9 * 2.0 * seq * hdim * inter * (mlp_calls // 2)
    achieved = mlp_flops / (mlp_ms / 1e3) / 1e12 if mlp_ms > 0 else None
    peak_tf = peaks["bf16_tflops_sustained"]
    roofline = {"bound": "tensor", "kernel": "bt::gemm::gemm_kernel_pair, tcgen05 cta_group::2 (6 launches per MLP block: gate|up fused, "
                                             "down (+ residual), dh->dgate/dup, dWd, dWg|dWu stacked, dx)",
                "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf if achieved else None,
                "peak_kind": f"{peak_kind} cuBLAS bf16, sustained (kernel timed inside a long step); burst {peaks['bf16_tflops']}",
                "frac_of_burst": achieved / peaks["bf16_tflops"] if achieved else None,
                "flops_per_launch": mlp_flops / gemm_launches if gemm_launches else None,
                "avg_launch_ms": mlp_ms / gemm_launches if gemm_launches else None, "launches_timed": gemm_launches,
                "traffic": 1.56e9, "traffic_note": "dram read+write bytes per launch, mean of the 6 launches of a block, ncu --set full "
                                                        "capture of bench.py --only-op mlp (profiles/gemm_kernel_pair_mlp_8192x4096x12288.md)"}

    line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_value / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"qwen3-8b ({args.layers} layers, hidden 4096, intermediate {args.intermediate}, vocab 151936) seq {seq} "
                                   "batch 1 fwd+bwd+AdamW, random init",
                       "global_batch_tokens": seq * world, "seq_len": seq,
                       "parallelism": parallelism,
                       "attention": "torch SDPA", "activation_checkpointing": bool(args.grad_checkpoint), "gemm_tiles": "dynamic" if dynamic_tiles else "fixed", "fused_layers": fused_layers, "gemm_projections": args.gemm_projections if fused_layers else "off", "optimizer": (("bastile_b200.optim.AdamW" + (", updates overlapped with the backward pass" if overlap_opt else "")) if args.optimizer == "bastile" else "torch.optim.AdamW(fused=True)")
                                    + ", bf16 params and state",
                       "l2": "each step streams ~65 GB of weights, gradients and optimizer state: far larger than the 126 MB L2"},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": seq * 8, "d2h_bytes_per_step": 4,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": launches, "clocks": clocks.summary(), "roofline": roofline, "loss": last_loss,
            "op_ms_per_step": {k: v[1] / args.steps for k, v in op_ms.items()},
            "peak_mem_GB": torch.cuda.max_memory_allocated() / 1e9, "applied": applied}

    if rank == 0:
        published = 12.0e3  # reference README bar chart, seq 8192 (intermediate 14336, other software stack)
        line["reference_published_tokens_per_s_seq8192"] = published
    if world == 1:
        del net, model, opt
        torch.cuda.empty_cache()
        if not args.no_per_op:
            try:
                line["per_op"] = per_op_bench(peaks)
            except Exception as exc:  # the headline number stands on its own
                line["per_op"] = {"error": repr(exc)}
            torch.cuda.empty_cache()
        if not args.no_cpu_baseline:
            v, times, threads = cpu_reference_sample(256)
            line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "reference",
                                    "sample": "HF transformers eager Qwen3 (unpatched), fp32, Qwen3-8B shapes at 256 tokens: "
                                              "36 x (decoder layer fwd+bwd) + (final norm + lm_head + cross-entropy fwd+bwd) "
                                              "+ AdamW scaled to 8.19 B parameters; "
                                              + json.dumps({k: round(v, 3) for k, v in times.items()})}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
