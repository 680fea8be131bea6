"""Generate the golden fixtures in this directory.  Run where the reference checkout
exists:  ``python tests/golden/make_golden.py <path-to-reference-checkout>``
(or set ``BASTILE_REFERENCE``).  The fixtures are what the tests read; this script is
kept so that they can be regenerated and audited.

Sources of truth, per fixture
  lce_*.npz        the reference's own fused loss, pure-torch vocabulary-chunked path
                   (fused_linear_cross_entropy(..., v_chunk_size=), src/bastile/ops/
                   fused_linear_cross_entropy.py:198-298, 304-399) executed on CPU fp32.
  patch_engine.json  the reference's apply()/get_patched_ops()/reset()/list_patches()
                   executed on CPU (src/bastile/core.py, registry.py).
  rmsnorm/rope/mlp_hf.npz  the HuggingFace eager modules the reference replaces
                   (transformers.models.qwen3.modeling_qwen3: Qwen3RMSNorm,
                   apply_rotary_pos_emb, Qwen3MLP) with torch autograd, CPU fp32 - what
                   the reference's unit tests compare with (tests/ops/test_*.py).
  tiny_qwen3.npz   loss and gradients of the tiny Qwen3ForCausalLM (2 layers, hidden
                   256, 4/2 heads, head_dim 64, intermediate 768, vocab 4096; batch 2 x
                   128, seed 0, 10 % labels = -100) in HF eager on CPU fp32.
"""

from __future__ import annotations

import json
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REF = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BASTILE_REFERENCE", "reference"))


def tiny_qwen3_inputs():
    """Deterministic inputs of the tiny-model case (also used by the tests)."""
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 4096, (2, 128), generator=g)
    mask = torch.rand(2, 128, generator=g) < 0.10
    labels = ids.clone()
    labels[mask] = -100
    return ids, labels


def tiny_qwen3_config():
    from transformers import Qwen3Config

    return Qwen3Config(vocab_size=4096, hidden_size=256, intermediate_size=768, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6,
                       rope_theta=1e6, tie_word_embeddings=False, max_position_embeddings=512,
                       attention_dropout=0.0, use_cache=False)


def build_tiny_qwen3(dtype=torch.float32):
    from transformers import Qwen3ForCausalLM

    torch.manual_seed(0)
    model = Qwen3ForCausalLM(tiny_qwen3_config()).to(dtype)
    model.train()
    return model


def main() -> None:
    sys.path.insert(0, str(REF / "src"))
    import bastile as ref  # the reference package
    from bastile.ops.fused_linear_cross_entropy import fused_linear_cross_entropy as ref_lce

    # ---- patch engine --------------------------------------------------------------
    import transformers.models.qwen3.modeling_qwen3 as q3
    import importlib

    eng = {}
    eng["list_patches_before_apply"] = ref.list_patches()
    eng["apply_default"] = ref.apply()
    eng["list_patches"] = ref.list_patches()
    eng["get_patched_ops_after_apply"] = ref.get_patched_ops()
    eng["apply_again"] = ref.apply()
    eng["reset_all"] = ref.reset()
    eng["get_patched_ops_after_reset"] = ref.get_patched_ops()
    importlib.reload(q3)
    eng["apply_only_rms"] = ref.apply(rms_norm=True, swiglu=False, rope=False, fused_linear_cross_entropy=False)
    eng["reset_named"] = ref.reset(["rms_norm_qwen3"])
    eng["apply_llama"] = ref.apply(model_type="llama")
    ref.reset()
    importlib.reload(q3)
    eng["apply_qwen3_no_lce"] = ref.apply(model_type="qwen3", fused_linear_cross_entropy=False)
    ref.reset()
    importlib.reload(q3)
    eng["version"] = ref.__version__
    eng["all"] = sorted(ref.__all__)
    (HERE / "patch_engine.json").write_text(json.dumps(eng, indent=1) + "\n")

    # ---- fused linear cross-entropy: the reference itself ----------------------------
    def lce_case(name, bt, h, v, seed, w_std, ignore_every=0, reduction="mean", three_d=False, all_ignored=False,
                 v_chunk=128, chunk=4096):
        torch.manual_seed(seed)
        x = (torch.randn(bt, h)).requires_grad_(True)
        w = (torch.randn(v, h) * w_std).requires_grad_(True)
        t = torch.randint(0, v, (bt,))
        if ignore_every:
            t[::ignore_every] = -100
        if all_ignored:
            t[:] = -100
        xin, tin = (x.view(2, bt // 2, h), t.view(2, bt // 2)) if three_d else (x, t)
        loss = ref_lce(xin, w, tin, ignore_index=-100, reduction=reduction, v_chunk_size=v_chunk, chunk_size=chunk)
        loss.backward()
        np.savez_compressed(HERE / f"lce_{name}.npz", x=x.detach().numpy(), w=w.detach().numpy(), t=t.numpy(),
                            loss=loss.detach().numpy(), dx=x.grad.numpy(), dw=w.grad.numpy(),
                            reduction=np.array(reduction), three_d=np.array(three_d))

    lce_case("loss_fp32", 32, 256, 1024, 42, 1.0)                    # tests/ops/test_fused_...py:18-34
    lce_case("grads", 16, 128, 512, 42, 1.0)                          # :58-88
    lce_case("ignore_index", 48, 128, 512, 42, 1.0, ignore_every=3)   # :91-113
    lce_case("three_d", 32, 128, 512, 42, 1.0, three_d=True)          # :116-136
    lce_case("sum", 24, 64, 384, 7, 0.5, ignore_every=5, reduction="sum")
    lce_case("all_ignored", 8, 64, 256, 3, 1.0, all_ignored=True)
    # One row chunk only: with more than one, the reference's vocabulary-chunked path
    # overwrites dW per row chunk instead of accumulating it (:294-296), so its dW is
    # only right when chunk_size >= rows.
    lce_case("ragged", 37, 72, 331, 11, 0.3, ignore_every=4, v_chunk=100)

    # ---- HF eager modules ---------------------------------------------------------------
    torch.manual_seed(1)
    norm = q3.Qwen3RMSNorm(192, eps=1e-6)
    with torch.no_grad():
        norm.weight.copy_(1 + 0.02 * torch.randn(192))
    x = torch.randn(3, 17, 192, requires_grad=True)
    dy = torch.randn(3, 17, 192)
    y = norm(x)
    y.backward(dy)
    np.savez_compressed(HERE / "rmsnorm_hf.npz", x=x.detach().numpy(), w=norm.weight.detach().numpy(), dy=dy.numpy(),
                        y=y.detach().numpy(), dx=x.grad.numpy(), dw=norm.weight.grad.numpy(), eps=np.float32(1e-6))

    torch.manual_seed(2)
    b, hq, hk, t, d = 2, 4, 2, 33, 64
    q = torch.randn(b, hq, t, d, requires_grad=True)
    k = torch.randn(b, hk, t, d, requires_grad=True)
    inv_freq = 1.0 / (1e6 ** (torch.arange(0, d, 2).float() / d))
    freqs = torch.outer(torch.arange(t).float(), inv_freq)
    emb = torch.cat((freqs, freqs), -1)
    cos, sin = emb.cos()[None], emb.sin()[None]
    qo, ko = q3.apply_rotary_pos_emb(q, k, cos, sin)
    dq, dk = torch.randn_like(qo), torch.randn_like(ko)
    torch.autograd.backward([qo, ko], [dq, dk])
    np.savez_compressed(HERE / "rope_hf.npz", q=q.detach().numpy(), k=k.detach().numpy(), cos=cos.numpy(),
                        sin=sin.numpy(), q_out=qo.detach().numpy(), k_out=ko.detach().numpy(), dq_out=dq.numpy(),
                        dk_out=dk.numpy(), dq=q.grad.numpy(), dk=k.grad.numpy())

    torch.manual_seed(3)
    cfg = tiny_qwen3_config()
    cfg.hidden_size, cfg.intermediate_size = 64, 160
    mlp = q3.Qwen3MLP(cfg)
    with torch.no_grad():
        for p in mlp.parameters():
            p.normal_(0, 0.1)
    x = torch.randn(21, 64, requires_grad=True)
    dy = torch.randn(21, 64)
    y = mlp(x)
    y.backward(dy)
    np.savez_compressed(HERE / "mlp_hf.npz", x=x.detach().numpy(), dy=dy.numpy(), wg=mlp.gate_proj.weight.detach().numpy(),
                        wu=mlp.up_proj.weight.detach().numpy(), wd=mlp.down_proj.weight.detach().numpy(),
                        y=y.detach().numpy(), dx=x.grad.numpy(), dwg=mlp.gate_proj.weight.grad.numpy(),
                        dwu=mlp.up_proj.weight.grad.numpy(), dwd=mlp.down_proj.weight.grad.numpy())

    # ---- tiny Qwen3 whole model, HF eager, CPU fp32 -------------------------------------------
    importlib.reload(q3)
    model = build_tiny_qwen3()
    ids, labels = tiny_qwen3_inputs()
    out = model(input_ids=ids, labels=labels)
    out.loss.backward()
    grads = {n: p.grad for n, p in model.named_parameters()}
    keep_full = ["model.norm.weight", "model.layers.0.input_layernorm.weight",
                 "model.layers.1.self_attn.q_norm.weight", "model.layers.1.self_attn.k_norm.weight",
                 "model.layers.0.post_attention_layernorm.weight"]
    payload = {"loss": out.loss.detach().numpy(), "ids": ids.numpy(), "labels": labels.numpy(),
               "names": np.array(list(grads)), "grad_norms": np.array([g.norm().item() for g in grads.values()], np.float64),
               "param_norms": np.array([p.norm().item() for p in model.parameters()], np.float64)}
    for n in keep_full:
        payload["grad::" + n] = grads[n].numpy()
    # a slice of a big gradient, enough to catch layout mistakes
    payload["grad::lm_head.weight[:64,:64]"] = grads["lm_head.weight"][:64, :64].numpy()
    payload["grad::model.layers.1.mlp.down_proj.weight[:64,:64]"] = grads["model.layers.1.mlp.down_proj.weight"][:64, :64].numpy()
    np.savez_compressed(HERE / "tiny_qwen3.npz", **payload)
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()
